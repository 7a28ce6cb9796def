// Runtime boundary mirrored from the reference: Resource / Resources (src/03runtime/include/runtime/resource.h:10-45),
// Routine and Node = RoutineWorkspace (src/03runtime/include/runtime/stream.h:10-22).  The `workspaceOffset`
// field carries the workspace SIZE in bytes when a kernel returns it from lower(), and the allocator later
// overwrites it with the offset into the stack, exactly as in the reference.
#pragma once
#include "common.h"
#include <functional>
#include <utility>
#include <unordered_map>

namespace refactor::runtime {

    class Resource {
    public:
        virtual ~Resource() = default;
        virtual size_t resourceTypeId() const = 0;
        virtual std::string_view description() const = 0;
        bool is(size_t id) const noexcept { return resourceTypeId() == id; }
    };
    using ResourceBox = std::unique_ptr<Resource>;

    class Resources {
        std::unordered_map<size_t, ResourceBox> _internal;

    public:
        Resource *fetch(size_t id) noexcept {
            auto it = _internal.find(id);
            return it == _internal.end() ? nullptr : it->second.get();
        }
        Resource *fetchOrStore(ResourceBox r) noexcept {
            auto [it, ok] = _internal.try_emplace(r->resourceTypeId(), std::move(r));
            (void) ok;
            return it->second.get();
        }
        Resource *fetchOrStore(size_t id, std::function<ResourceBox()> f) {
            auto it = _internal.find(id);
            if (it == _internal.end()) it = _internal.emplace(id, f()).first;
            return it->second.get();
        }
        template<class T> T *fetch() noexcept { return dynamic_cast<T *>(fetch(T::typeId())); }
        template<class T, class... Args> T *fetchOrStore(Args &&...args) {
            return dynamic_cast<T *>(fetchOrStore(T::typeId(), [&]() -> ResourceBox { return T::build(std::forward<Args>(args)...); }));
        }
    };

    using Routine = std::function<void(Resources &, void *, void const *const *, void *const *)>;
    inline void emptyRoutine(Resources &, void *, void const *const *, void *const *) {}

    struct Node {
        Routine routine;
        size_t workspaceOffset;
        template<class T> Node(T &&r, size_t wso = 0) noexcept : routine(std::forward<T>(r)), workspaceOffset(wso) {}
    };

    // The CUDA stream every routine of one Stream launches on.  The reference launches on the legacy default
    // stream; a dedicated stream is what makes CUDA-graph capture of a whole step possible.
    class CudaStream final : public Resource {
    public:
        void *stream;// cudaStream_t
        explicit CudaStream(void *s) : stream(s) {}
        ~CudaStream() override;
        static size_t typeId() noexcept;
        static ResourceBox build();
        size_t resourceTypeId() const noexcept override { return typeId(); }
        std::string_view description() const noexcept override { return "CUDA stream of this runtime::Stream"; }
    };

}// namespace refactor::runtime
