// Python surface, same names as the reference's module (src/09python_ffi/src/main.cpp:23-56):
//   find_device, config_log, _make_operator, _make_tensor, _make_data, _make_data_ex, _make_compiler,
//   Compiler.{substitute, set_input, set_input_info, check_variables, zero_inputs, get_tensor, compile, compile_on, serialize},
//   Executor.{dispatch, set_input, set_input_blob, get_output, get_output_blob, run, bench, trace, dbg}.
//   compile("cuda", ...) lowers every node to a B200 kernel; any other target has no kernels here and fails with
//   "No kernel selected for ...".  `passes`: "ce" and "lp" are accepted for compatibility (there are no symbolic shapes to
//   evaluate and no NCHW operators to permute on this path); "fuse" runs the kernel-fusion rewrites, "fuse-step" also turns a
//   completely fused batch-1 greedy decode step into the single persistent kernel.
#include "rg/graph.h"
#include "rg/kv_blocks.h"
#include <cstring>
#include <cuda_runtime_api.h>
#include <filesystem>
#include <fstream>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <optional>
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

    // hardware::Device of the reference (src/02hardware/include/hardware/device.h), reduced to what this path needs: the
    // kind, the card, and — for tensor-parallel graphs — the communicator of this rank, which compile_on / dispatch store
    // in the Stream's Resources the way the reference's all-reduce test stores its NcclCommunicator
    // (src/04kernel/test/kernels/all_reduce/test_allreduce_nccl.cpp:24).
    struct Device {
        kernel::Target type;
        int card;
        uintptr_t comm = 0;
        int world = 1, rank = 0;
        void setContext() const {
            if (type == kernel::Target::Nvidia && cudaSetDevice(card) != cudaSuccess) RUNTIME_ERROR("cudaSetDevice(" + std::to_string(card) + ") failed");
        }
    };
    Arc<Device> findDevice(std::string type, int card) {
        std::transform(type.begin(), type.end(), type.begin(), ::tolower);
        auto d = std::make_shared<Device>();
        d->card = card;
        if (type == "cpu") d->type = kernel::Target::Cpu;
        else if (type == "nvidia" || type == "cuda") {
            d->type = kernel::Target::Nvidia;
            int n = 0;
            if (cudaGetDeviceCount(&n) != cudaSuccess || card < 0 || card >= n) RUNTIME_ERROR("find_device: no Nvidia card " + std::to_string(card));
        } else
            RUNTIME_ERROR("Unknown device type: \"" + type + "\"");
        return d;
    }

    // A tensor that stays on the device: what get_output_blob returns and set_input_blob accepts (Device::Blob, the
    // class the reference exposes as "Pinned").  It shares ownership of the stream whose memory it points into.
    struct DeviceBlob {
        std::shared_ptr<runtime::Stream> owner;
        void *ptr;
        size_t bytes;
        int device;
    };

    void writeNpy(std::ofstream os, char const *ptr, size_t size, DataType dt, std::vector<dim_t> const &shape) {
        // src/09python_ffi/src/executor.cc:144-183: version 1.0 header padded to 64 bytes; bf16 has no numpy type and is
        // written as raw 16-bit words
        std::string dims;
        for (auto d : shape) dims += std::to_string(d) + ",";
        char const *descr = "<f4";
        switch (dt) {
            case DataType::F32: descr = "<f4"; break;
            case DataType::U8: descr = "|u1"; break;
            case DataType::I8: descr = "|i1"; break;
            case DataType::U16: case DataType::BF16: descr = "<u2"; break;
            case DataType::I16: descr = "<i2"; break;
            case DataType::I32: descr = "<i4"; break;
            case DataType::I64: descr = "<i8"; break;
            case DataType::Bool: descr = "|b1"; break;
            case DataType::FP16: descr = "<f2"; break;
            case DataType::F64: descr = "<f8"; break;
            case DataType::U32: descr = "<u4"; break;
            case DataType::U64: descr = "<u8"; break;
            default: RUNTIME_ERROR("trace: data type has no npy descriptor");
        }
        std::string dict = std::string("{'descr': '") + descr + "', 'fortran_order': False, 'shape': (" + dims + "), }";
        const size_t aligned = (dict.size() + 11 + 63) & ~size_t(63);
        std::vector<char> header(aligned, ' ');
        static constexpr char MAGIC[]{static_cast<char>(0x93), 'N', 'U', 'M', 'P', 'Y', 1, 0};
        std::memcpy(header.data(), MAGIC, sizeof(MAGIC));
        const size_t len = aligned - 10;
        header[8] = static_cast<char>(len), header[9] = static_cast<char>(len >> 8);
        std::memcpy(header.data() + 10, dict.data(), dict.size());
        header[aligned - 1] = '\n';
        os.write(header.data(), static_cast<std::streamsize>(aligned));
        os.write(ptr, static_cast<std::streamsize>(size));
    }
    void writeText(std::ofstream os, char const *ptr, size_t size, DataType dt, std::vector<dim_t> const &shape) {
        os << dt.name() << '<';
        for (size_t i = 0; i < shape.size(); ++i) os << (i ? "x" : "") << shape[i];
        os << '>' << std::endl;
        auto dump = [&](auto const *p, size_t n) {
            for (size_t i = 0; i < n; ++i) os << +p[i] << '\t';
        };
        switch (dt) {
            case DataType::F32: dump(reinterpret_cast<float const *>(ptr), size / 4); break;
            case DataType::F64: dump(reinterpret_cast<double const *>(ptr), size / 8); break;
            case DataType::I32: dump(reinterpret_cast<int32_t const *>(ptr), size / 4); break;
            case DataType::I64: dump(reinterpret_cast<int64_t const *>(ptr), size / 8); break;
            case DataType::U32: dump(reinterpret_cast<uint32_t const *>(ptr), size / 4); break;
            case DataType::U64: dump(reinterpret_cast<uint64_t const *>(ptr), size / 8); break;
            case DataType::U8: case DataType::Bool: dump(reinterpret_cast<uint8_t const *>(ptr), size); break;
            case DataType::I8: dump(reinterpret_cast<int8_t const *>(ptr), size); break;
            default: dump(reinterpret_cast<uint16_t const *>(ptr), size / 2); break;// 16-bit types as raw words
        }
    }

    class Executor {
        Arc<computation::Graph> _graph;// kept for dispatch (re-lowering on another device)
        std::shared_ptr<runtime::Stream> _stream;
        std::vector<Arc<Tensor>> _inputs, _outputs;

    public:
        Executor(Arc<computation::Graph> g, std::shared_ptr<runtime::Stream> s, std::vector<Arc<Tensor>> in, std::vector<Arc<Tensor>> out)
            : _graph(std::move(g)), _stream(std::move(s)), _inputs(std::move(in)), _outputs(std::move(out)) {}
        static std::shared_ptr<runtime::Stream> lowerOn(computation::Graph const &g, Device const &device, std::string const &allocator,
                                                        std::vector<Arc<Tensor>> *in, std::vector<Arc<Tensor>> *out) {
            device.setContext();
            auto kg = g.lower(device.type);
            if (in) {
                in->clear();
                for (auto e : kg.globalInputs) in->push_back(kg.edges[e].tensor);
            }
            if (out) *out = kg.outputTensors;
            std::shared_ptr<runtime::Stream> stream = kg.lower(allocator);
            if (device.comm) stream->resources().fetchOrStore(kernel::makeCommResource(reinterpret_cast<void *>(device.comm)));
            return stream;
        }
        // src/09python_ffi/src/executor.cc:16-33: lower the graph again for `device`, carry the current input data over
        void dispatch(Arc<Device> device, std::string allocator) {
            ASSERT(device, "dispatch: no device");
            auto fresh = lowerOn(*_graph, *device, allocator, nullptr, nullptr);
            std::vector<uint8_t> buffer;
            for (count_t i = 0; i < _inputs.size(); ++i) {
                const size_t bytes = _stream->edgeBytes(true, i);
                buffer.resize(bytes);
                _stream->bind();
                if (cudaMemcpy(buffer.data(), _stream->inputAddress(i), bytes, cudaMemcpyDeviceToHost) != cudaSuccess) RUNTIME_ERROR("dispatch: read-back failed");
                fresh->setData(i, buffer.data(), bytes);
                fresh->sync();
            }
            _stream = std::move(fresh);
        }
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
        void setInputFromBlob(count_t i, Arc<DeviceBlob> blob) {
            ASSERT(blob && i < _inputs.size(), "set_input_blob: bad argument");
            ASSERT(blob->bytes == _stream->edgeBytes(true, i), "input size mismatch");
            if (blob->device == _stream->device()) {
                setInputBlob(i, reinterpret_cast<uintptr_t>(blob->ptr), blob->bytes);
            } else {
                _stream->deviceSync();
                if (cudaMemcpyPeer(_stream->inputAddress(i), _stream->device(), blob->ptr, blob->device, blob->bytes) != cudaSuccess)
                    RUNTIME_ERROR("set_input_blob: peer copy failed");
            }
        }
        // src/09python_ffi/src/executor.cc:61-64: the output stays on the device
        Arc<DeviceBlob> getOutputBlob(count_t i) const {
            ASSERT(i < _outputs.size(), "output index out of range");
            _stream->sync();
            return std::make_shared<DeviceBlob>(DeviceBlob{_stream, _stream->outputAddress(i), _stream->edgeBytes(false, i), _stream->device()});
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
        // src/09python_ffi/src/executor.cc:186-248: runs the graph node by node and dumps every input and output tensor of every
        // node as <path>/data<NNNNNN>.<format> (format "npy", "text", or anything else for raw bytes) with a node<NNNNNN>.meta
        // listing per node: "node <i> <name>", then "input|output <k> <edge name> <file>" lines.
        void trace(std::string path_, std::string format) {
            namespace fs = std::filesystem;
            auto path = fs::path(std::move(path_));
            fs::create_directories(path);
            ASSERT(fs::is_directory(path), "Failed to create \"" + path.string() + "\"");
            size_t dataIdx = 0;
            std::vector<char> buffer;
            auto numbered = [](char const *prefix, size_t n, std::string const &ext) {
                char buf[64];
                std::snprintf(buf, sizeof(buf), "%s%06zu.", prefix, n);
                return std::string(buf) + ext;
            };
            _stream->trace([&](count_t nodeIdx, void const *const *inputs, void const *const *outputs) {
                auto const &node = _stream->node(nodeIdx);
                std::ostringstream meta;
                auto dump = [&](size_t edgeIdx, void const *address) -> std::string {
                    auto const &edge = _stream->edge(edgeIdx);
                    if (!address || !edge.bytes) return "";
                    buffer.resize(edge.bytes);
                    if (cudaMemcpy(buffer.data(), address, edge.bytes, cudaMemcpyDeviceToHost) != cudaSuccess) RUNTIME_ERROR("trace: copy failed");
                    auto file = path / numbered("data", dataIdx++, format);
                    fs::remove(file);
                    std::ofstream os(file, std::ios::binary);
                    if (format == "npy") writeNpy(std::move(os), buffer.data(), edge.bytes, edge.dataType, edge.shape);
                    else if (format == "text")
                        writeText(std::move(os), buffer.data(), edge.bytes, edge.dataType, edge.shape);
                    else
                        os.write(buffer.data(), static_cast<std::streamsize>(edge.bytes));
                    return file.string();
                };
                meta << "node\t" << nodeIdx << '\t' << node.name << std::endl;
                for (size_t i = 0; i < node.inputs.size(); ++i)
                    meta << "input\t" << i << '\t' << _stream->edge(node.inputs[i]).name << '\t' << dump(node.inputs[i], inputs[i]) << std::endl;
                for (size_t i = 0; i < node.outputs.size(); ++i)
                    meta << "output\t" << i << '\t' << _stream->edge(node.outputs[i]).name << '\t' << dump(node.outputs[i], outputs[i]) << std::endl;
                std::ofstream(path / numbered("node", nodeIdx, "meta")) << meta.str();
            });
        }
        // src/09python_ffi/src/executor.cc:250-255: one line per node
        void debugInfo() const {
            for (size_t i = 0; i < _stream->nodeCount(); ++i) py::print(py::str("{}. {}").format(i, std::string(_stream->nodeName(i))));
        }
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

        std::vector<py::ssize_t> static shapeOf(Tensor const &t) { return std::vector<py::ssize_t>(t.shape.begin(), t.shape.end()); }

    public:
        explicit Compiler(computation::Graph g) : _g(std::move(g)) {}
        // shapes are concrete in every graph this module builds: there is nothing to substitute
        void substitute(char const *name, int64_t) { py::print(py::str("WARNING: variable \"{}\" not exist").format(name)); }
        void setInput(size_t i, py::array data) {
            ASSERT(i < _g.globalInputs.size(), "input index out of range");
            std::vector<dim_t> shape(data.shape(), data.shape() + data.ndim());
            _g.edges[_g.globalInputs[i]].tensor = Tensor::share(parseNumpy(data.dtype()), shape);
        }
        void setInputInfo(size_t i, int dataType, std::vector<int64_t> dims) {
            ASSERT(i < _g.globalInputs.size(), "input index out of range");
            _g.edges[_g.globalInputs[i]].tensor = Tensor::share(*DataType::parse(dataType), std::vector<dim_t>(dims.begin(), dims.end()));
        }
        // src/09python_ffi/src/compiler.cc:44-45: names of unresolved symbolic variables — none can exist here; shapes are inferred
        std::vector<std::string> checkVariables(bool) {
            _g.inferShapes();
            return {};
        }
        std::vector<py::array> zeroInputs() const {
            std::vector<py::array> ans;
            for (auto e : _g.globalInputs) {
                auto const &t = *_g.edges[e].tensor;
                py::array a(numpyOf(t.dataType), shapeOf(t));
                std::memset(a.mutable_data(), 0, static_cast<size_t>(a.nbytes()));
                ans.push_back(std::move(a));
            }
            return ans;
        }
        std::optional<py::array> getTensor(char const *name) const {
            for (auto const &e : _g.edges)
                if (e.name == name && e.tensor) {
                    py::array a(numpyOf(e.tensor->dataType), shapeOf(*e.tensor));
                    if (e.tensor->data && e.tensor->data->bytes.size() == static_cast<size_t>(a.nbytes())) std::memcpy(a.mutable_data(), e.tensor->data->bytes.data(), a.nbytes());
                    return a;
                }
            return std::nullopt;
        }
        // src/09python_ffi/src/compiler.cc:47-88
        Arc<Executor> compileOn(Arc<Device> device, std::string allocator, std::vector<std::string> passes) {
            ASSERT(device, "compile_on: no device");
            _g.inferShapes();
            bool fuse = false, step = false;
            for (auto const &p : passes) {
                if (p == "fuse") fuse = true;
                if (p == "fuse-step") fuse = step = true;
            }
            auto graph = std::make_shared<computation::Graph>(cloneGraph());
            if (fuse) graph->fuse(step);
            std::vector<Arc<Tensor>> in, out;
            auto stream = Executor::lowerOn(*graph, *device, allocator, &in, &out);
            return std::make_shared<Executor>(std::move(graph), std::move(stream), std::move(in), std::move(out));
        }
        Arc<Executor> compile(std::string target, std::string allocator, std::vector<std::string> passes) {
            std::transform(target.begin(), target.end(), target.begin(), ::tolower);
            auto device = std::make_shared<Device>();
            if (target == "cuda" || target == "nvidia") {
                device->type = kernel::Target::Nvidia;
                if (cudaGetDevice(&device->card) != cudaSuccess) device->card = 0;// the calling thread's current GPU
            } else if (target == "cpu") {
                device->type = kernel::Target::Cpu, device->card = 0;
            } else
                RUNTIME_ERROR("Unknown target: " + target);
            return compileOn(std::move(device), std::move(allocator), std::move(passes));
        }
        // operator names of the graph after the given passes, in execution order (what compile would lower)
        std::vector<std::string> plan(std::vector<std::string> passes) {
            _g.inferShapes();
            auto graph = cloneGraph();
            bool fuse = false, step = false;
            for (auto const &p : passes) {
                if (p == "fuse") fuse = true;
                if (p == "fuse-step") fuse = step = true;
            }
            if (fuse) graph.fuse(step);
            std::vector<std::string> ans;
            for (auto const &n : graph.nodes)
                if (!n.op->isIdentity()) ans.emplace_back(n.op->name());
            return ans;
        }
        // src/09python_ffi/src/compiler.cc:140-169: <path>/graph.info (text) and <path>/graph.data (constants)
        void serialize(std::string path_) {
            namespace fs = std::filesystem;
            _g.inferShapes();
            auto path = fs::path(std::move(path_));
            fs::create_directories(path);
            ASSERT(fs::is_directory(path), "Failed to create \"" + path.string() + "\"");
            auto [text, data] = _g.serialize();
            std::ofstream(path / "graph.info") << text;
            std::ofstream(path / "graph.data", std::ios::binary).write(reinterpret_cast<char const *>(data.data()), static_cast<std::streamsize>(data.size()));
        }

    private:
        // operators are immutable once built, so a copy of the graph shares nothing that a rewrite could disturb except the
        // operator boxes, which are rebuilt from the originals' type names by the caller-visible makeOperator path
        computation::Graph cloneGraph() const {
            computation::Graph c;
            c.edges = _g.edges;
            c.globalInputs = _g.globalInputs, c.globalOutputs = _g.globalOutputs;
            for (auto const &n : _g.nodes) {
                computation::Graph::Node m;
                m.op = n.op->clone();
                m.name = n.name, m.inputs = n.inputs, m.outputs = n.outputs;
                c.nodes.push_back(std::move(m));
            }
            return c;
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

    // src/09python_ffi/src/import.cpp:40-55: a constant whose bytes live in an external file (ONNX external data)
    Arc<Tensor> makeTensorWithExternalData(int dataType, std::vector<int64_t> shape, std::string file, int64_t offset) {
        auto dt = DataType::parse(static_cast<uint8_t>(dataType));
        ASSERT(dt.has_value(), "unknown data type code");
        auto t = Tensor::share(*dt, std::vector<dim_t>(shape.begin(), shape.end()));
        std::ifstream stream(file, std::ios::binary);
        ASSERT(stream.is_open(), "No such file: \"" + file + "\"");
        stream.seekg(offset);
        stream.read(static_cast<char *>(t->malloc()), static_cast<std::streamsize>(t->bytesSize()));
        ASSERT(static_cast<size_t>(stream.gcount()) == t->bytesSize(), "external data file \"" + file + "\" is shorter than the tensor");
        return t;
    }
    // src/09python_ffi/src/main.cpp:27 config_log: the reference routes fmtlog to a file; this layer logs nothing, so the
    // call only validates its arguments
    void configLog(std::string, std::string level) {
        for (auto const *ok : {"DBG", "INF", "WRN", "ERR", "OFF", "dbg", "inf", "wrn", "err", "off"})
            if (level == ok) return;
        RUNTIME_ERROR("config_log: unknown level " + level);
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
    py::class_<Device, Arc<Device>>(m, "Device")
        .def_property_readonly("card", [](Device const &d) { return d.card; })
        .def_property_readonly("kind", [](Device const &d) { return d.type == kernel::Target::Nvidia ? "nvidia" : "cpu"; })
        // tensor parallelism: this rank's communicator (address of an rg_comm, kept alive by the caller) travels with the device
        .def("set_communicator", [](Device &d, uintptr_t comm, int world, int rank) { d.comm = comm, d.world = world, d.rank = rank; },
             py::arg("comm"), py::arg("world") = 1, py::arg("rank") = 0);
    py::class_<DeviceBlob, Arc<DeviceBlob>>(m, "Pinned")
        .def_property_readonly("address", [](DeviceBlob const &b) { return reinterpret_cast<uintptr_t>(b.ptr); })
        .def_property_readonly("size", [](DeviceBlob const &b) { return b.bytes; })
        .def_property_readonly("device", [](DeviceBlob const &b) { return b.device; });
    m.def("config_log", &configLog)
        .def("find_device", &findDevice)
        .def("_make_operator", &makeOp)
        .def("_make_tensor", &makeTensor)
        .def("_make_data", &makeTensorWithData, py::arg("data"), py::arg("data_type") = 0)
        .def("_make_data_ex", &makeTensorWithExternalData)
        .def("_make_compiler", &makeCompiler);
    // paged-KV block allocator (host side): tables and lengths come back as numpy arrays ready for Executor.set_input
    using runtime::KvBlockAllocator;
    py::class_<KvBlockAllocator>(m, "KvBlockAllocator")
        .def(py::init<uint32_t, uint32_t, uint32_t, uint32_t>(), py::arg("n_blocks"), py::arg("page_size"), py::arg("max_seqs"), py::arg("max_blocks_per_seq"))
        .def("add_sequence", &KvBlockAllocator::addSequence, py::arg("id"), py::arg("tokens"))
        .def("append", &KvBlockAllocator::append, py::arg("id"), py::arg("n") = 1)
        .def("release", &KvBlockAllocator::release)
        .def("length", &KvBlockAllocator::length)
        .def("row", &KvBlockAllocator::row)
        .def("blocks", &KvBlockAllocator::blocks)
        .def_property_readonly("free_blocks", &KvBlockAllocator::freeBlocks)
        .def("table", [](KvBlockAllocator const &a) {
            py::array_t<int32_t> t({static_cast<py::ssize_t>(a.maxSeqs()), static_cast<py::ssize_t>(a.maxBlocksPerSeq())});
            std::memcpy(t.mutable_data(), a.table().data(), a.table().size() * sizeof(int32_t));
            return t;
        })
        .def("lengths", [](KvBlockAllocator const &a) {
            auto v = a.lengths();
            py::array_t<int64_t> t(static_cast<py::ssize_t>(v.size()));
            std::memcpy(t.mutable_data(), v.data(), v.size() * sizeof(int64_t));
            return t;
        });
    py::class_<Compiler, Arc<Compiler>>(m, "Compiler")
        .def("substitute", &Compiler::substitute)
        .def("set_input", &Compiler::setInput)
        .def("set_input_info", &Compiler::setInputInfo)
        .def("check_variables", &Compiler::checkVariables)
        .def("zero_inputs", &Compiler::zeroInputs)
        .def("get_tensor", &Compiler::getTensor)
        .def("compile", &Compiler::compile)
        .def("compile_on", &Compiler::compileOn)
        .def("plan", &Compiler::plan)
        .def("serialize", &Compiler::serialize);
    py::class_<Executor, Arc<Executor>>(m, "Executor")
        .def("dispatch", &Executor::dispatch)
        .def("set_input", &Executor::setInput)
        .def("set_input_blob", &Executor::setInputBlob)
        .def("set_input_blob", &Executor::setInputFromBlob)
        .def("set_input_async", &Executor::setInputAsync)
        .def("get_output_into", &Executor::getOutputAsync)
        .def("get_output", &Executor::getOutput)
        .def("get_output_blob", &Executor::getOutputBlob)
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
