// kernel::Graph::lower and runtime::Stream (see rg/graph.h).
#include "rg/graph.h"
#include <algorithm>
#include <cuda_runtime_api.h>

namespace refactor::kernel {
    static size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

    std::unique_ptr<runtime::Stream> Graph::lower(std::string const &allocator) const {
        constexpr size_t ALIGN = 256;
        runtime::Resources res;
        std::vector<runtime::Stream::NodeSlot> ns;
        std::vector<size_t> wsBytes;
        for (auto const &n : nodes) {
            auto rw = n.kernel->lower(res);
            wsBytes.push_back(rw.workspaceOffset);
            ns.push_back({std::move(rw.routine), 0, n.inputs, n.outputs, n.name});
        }
        // which edges live on the stack: everything that is not a constant, a global input or a global output
        std::vector<char> own(edges.size(), 0);
        for (auto e : globalInputs) own[e] = 1;
        for (auto e : globalOutputs) own[e] = 1;
        for (size_t i = 0; i < edges.size(); ++i)
            if (edges[i].tensor && edges[i].tensor->data) own[i] = 1;
        std::vector<size_t> offset(edges.size(), 0);
        size_t stack = 0;
        if (allocator == "flat") {
            for (size_t i = 0; i < edges.size(); ++i)
                if (!own[i] && edges[i].tensor) offset[i] = stack, stack += alignUp(edges[i].tensor->bytesSize(), ALIGN);
            for (size_t i = 0; i < ns.size(); ++i) ns[i].workspaceOffset = stack, stack += alignUp(wsBytes[i], ALIGN);
        } else {
            // lifetime-based reuse: an edge's region is free after its last reader; first fit over the free list.
            // Workspaces with arrival counters need persistent zeroed memory, so they keep private regions.
            std::vector<size_t> last(edges.size(), 0);
            for (size_t n = 0; n < ns.size(); ++n)
                for (auto e : ns[n].inputs) last[e] = std::max(last[e], n);
            struct Free {
                size_t off, bytes;
            };
            std::vector<Free> freeList;
            std::vector<std::vector<size_t>> dying(ns.size());
            for (size_t e = 0; e < edges.size(); ++e)
                if (!own[e] && edges[e].tensor) dying[last[e]].push_back(e);
            for (size_t n = 0; n < ns.size(); ++n) {
                for (auto e : ns[n].outputs) {
                    if (own[e] || !edges[e].tensor) continue;
                    const size_t need = alignUp(edges[e].tensor->bytesSize(), ALIGN);
                    auto it = std::find_if(freeList.begin(), freeList.end(), [&](Free const &f) { return f.bytes >= need; });
                    if (it != freeList.end()) {
                        offset[e] = it->off;
                        if (it->bytes == need) freeList.erase(it);
                        else
                            it->off += need, it->bytes -= need;
                    } else {
                        offset[e] = stack, stack += need;
                    }
                }
                for (auto e : dying[n]) {
                    bool produced = false;
                    for (size_t m = 0; m <= n && !produced; ++m)
                        produced = std::find(ns[m].outputs.begin(), ns[m].outputs.end(), e) != ns[m].outputs.end();
                    if (produced) freeList.push_back({offset[e], alignUp(edges[e].tensor->bytesSize(), ALIGN)});
                }
            }
            for (size_t i = 0; i < ns.size(); ++i) ns[i].workspaceOffset = stack, stack += alignUp(wsBytes[i], ALIGN);
        }
        std::vector<runtime::Stream::EdgeSlot> es;
        for (size_t i = 0; i < edges.size(); ++i) {
            runtime::Stream::EdgeSlot slot{nullptr, offset[i], edges[i].tensor ? edges[i].tensor->bytesSize() : 0, edges[i].name};
            if (edges[i].tensor) slot.dataType = edges[i].tensor->dataType, slot.shape = edges[i].tensor->shape;
            if (own[i] && slot.bytes) {
                if (cudaMalloc(&slot.blob, slot.bytes) != cudaSuccess) RUNTIME_ERROR("cudaMalloc failed for edge " + edges[i].name);
                if (edges[i].tensor->data) {
                    if (cudaMemcpy(slot.blob, edges[i].tensor->data->bytes.data(), slot.bytes, cudaMemcpyHostToDevice) != cudaSuccess)
                        RUNTIME_ERROR("weight upload failed for edge " + edges[i].name);
                } else {
                    cudaMemset(slot.blob, 0, slot.bytes);
                }
            }
            es.push_back(std::move(slot));
        }
        return std::make_unique<runtime::Stream>(std::move(res), stack, std::move(ns), std::move(es), globalInputs, globalOutputs);
    }
}// namespace refactor::kernel

namespace refactor::runtime {
    static cudaStream_t streamOf(Resources &res) { return static_cast<cudaStream_t>(res.fetchOrStore<CudaStream>()->stream); }

    Stream::Stream(Resources res, size_t stackBytes, std::vector<NodeSlot> nodes, std::vector<EdgeSlot> edges,
                   std::vector<size_t> globalInputs, std::vector<size_t> globalOutputs)
        : _resources(std::move(res)), _stack(nullptr), _stackBytes(stackBytes), _nodes(std::move(nodes)),
          _edges(std::move(edges)), _globalInputs(std::move(globalInputs)), _globalOutputs(std::move(globalOutputs)),
          _graphExec(nullptr), _useGraph(true), _warm(false), _device(0) {
        cudaGetDevice(&_device);
        if (_stackBytes) {
            if (cudaMalloc(&_stack, _stackBytes) != cudaSuccess) RUNTIME_ERROR("cudaMalloc failed for the activation stack");
            cudaMemset(_stack, 0, _stackBytes);// workspaces with arrival counters start at zero
        }
        cudaDeviceSynchronize();
    }
    void Stream::bind() const {
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess || cur != _device)
            if (cudaSetDevice(_device) != cudaSuccess) RUNTIME_ERROR("cudaSetDevice failed");
    }
    Stream::~Stream() {
        cudaSetDevice(_device);
        cudaDeviceSynchronize();
        if (_graphExec) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(_graphExec));
        for (auto &e : _edges)
            if (e.blob) cudaFree(e.blob);
        if (_stack) cudaFree(_stack);
    }
    void *Stream::address(size_t e) const {
        return _edges[e].blob ? _edges[e].blob : static_cast<uint8_t *>(_stack) + _edges[e].stackOffset;
    }
    size_t Stream::edgeBytes(bool input, count_t i) const { return _edges[(input ? _globalInputs : _globalOutputs).at(i)].bytes; }
    void *Stream::inputAddress(count_t i) const { return address(_globalInputs.at(i)); }
    void *Stream::outputAddress(count_t i) const { return address(_globalOutputs.at(i)); }

    void Stream::setData(count_t i, void const *host, size_t bytes) {
        bind();
        auto &e = _edges[_globalInputs.at(i)];
        ASSERT(bytes == e.bytes, "setData: size of input " + e.name + " does not match its tensor");
        if (cudaMemcpyAsync(e.blob, host, bytes, cudaMemcpyHostToDevice, streamOf(_resources)) != cudaSuccess)
            RUNTIME_ERROR("setData: copy failed");
    }
    void Stream::setDataDevice(count_t i, void const *device, size_t bytes) {
        bind();
        auto &e = _edges[_globalInputs.at(i)];
        ASSERT(bytes == e.bytes, "setDataDevice: size of input " + e.name + " does not match its tensor");
        if (cudaMemcpyAsync(e.blob, device, bytes, cudaMemcpyDeviceToDevice, streamOf(_resources)) != cudaSuccess)
            RUNTIME_ERROR("setDataDevice: copy failed");
    }
    bool Stream::copyData(count_t i, void *host, size_t bytes) const {
        bind();
        auto const &e = _edges[_globalOutputs.at(i)];
        if (bytes != e.bytes) return false;
        auto st = streamOf(const_cast<Resources &>(_resources));
        if (cudaMemcpyAsync(host, address(_globalOutputs[i]), bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
        return cudaStreamSynchronize(st) == cudaSuccess;
    }
    void Stream::sync() const {
        bind();
        if (cudaStreamSynchronize(streamOf(const_cast<Resources &>(_resources))) != cudaSuccess) RUNTIME_ERROR("stream synchronize failed");
    }

    void Stream::deviceSync() const {
        bind();
        if (cudaDeviceSynchronize() != cudaSuccess) RUNTIME_ERROR("device synchronize failed");
    }

    void Stream::runEager() {
        std::vector<void const *> in;
        std::vector<void *> out;
        for (auto &n : _nodes) {
            in.clear(), out.clear();
            for (auto e : n.inputs) in.push_back(address(e));
            for (auto e : n.outputs) out.push_back(address(e));
            n.routine(_resources, static_cast<uint8_t *>(_stack) + n.workspaceOffset, in.data(), out.data());
        }
    }

    // First call: eager (loads kernels, sets function attributes).  Second call: the same host loop under stream
    // capture, instantiated as a CUDA graph.  Later calls: one cudaGraphLaunch.  All device addresses are fixed at
    // lower time and setData copies into existing blobs, so the captured graph stays valid.
    void Stream::run() {
        bind();
        auto st = streamOf(_resources);
        if (!_useGraph || !_warm) {
            runEager();
            _warm = true;
            return;
        }
        if (!_graphExec) {
            cudaGraph_t graph = nullptr;
            if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) RUNTIME_ERROR("stream capture failed to start");
            try {
                runEager();
            } catch (...) {
                cudaStreamEndCapture(st, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            if (cudaStreamEndCapture(st, &graph) != cudaSuccess || !graph) RUNTIME_ERROR("stream capture failed");
            cudaGraphExec_t exec = nullptr;
            const auto rc = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (rc != cudaSuccess) RUNTIME_ERROR("cudaGraphInstantiate failed");
            _graphExec = exec;
        }
        if (cudaGraphLaunch(static_cast<cudaGraphExec_t>(_graphExec), st) != cudaSuccess) RUNTIME_ERROR("cudaGraphLaunch failed");
    }

    // src/03runtime/src/stream.cc:71-86: per-node wall time, optionally synchronising after each node
    std::vector<std::chrono::nanoseconds> Stream::bench(bool sync_) {
        bind();
        std::vector<std::chrono::nanoseconds> ans;
        std::vector<void const *> in;
        std::vector<void *> out;
        auto st = streamOf(_resources);
        cudaStreamSynchronize(st);
        for (auto &n : _nodes) {
            in.clear(), out.clear();
            for (auto e : n.inputs) in.push_back(address(e));
            for (auto e : n.outputs) out.push_back(address(e));
            const auto t0 = std::chrono::steady_clock::now();
            n.routine(_resources, static_cast<uint8_t *>(_stack) + n.workspaceOffset, in.data(), out.data());
            if (sync_) cudaStreamSynchronize(st);
            ans.push_back(std::chrono::steady_clock::now() - t0);
        }
        cudaStreamSynchronize(st);
        return ans;
    }

    // src/03runtime/src/stream.cc:88-98: callback after every node with its input/output device addresses
    void Stream::trace(std::function<void(count_t, void const *const *, void const *const *)> cb) {
        bind();
        std::vector<void const *> in, outc;
        std::vector<void *> out;
        auto st = streamOf(_resources);
        for (count_t i = 0; i < _nodes.size(); ++i) {
            auto &n = _nodes[i];
            in.clear(), out.clear(), outc.clear();
            for (auto e : n.inputs) in.push_back(address(e));
            for (auto e : n.outputs) out.push_back(address(e)), outc.push_back(address(e));
            n.routine(_resources, static_cast<uint8_t *>(_stack) + n.workspaceOffset, in.data(), out.data());
            cudaStreamSynchronize(st);
            cb(i, in.data(), outc.data());
        }
    }
}// namespace refactor::runtime
