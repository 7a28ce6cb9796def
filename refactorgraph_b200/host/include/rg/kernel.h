// The drop-in boundary mirrored from the reference:
//   kernel::Tensor          src/04kernel/include/kernel/tensor.h:13-33
//   kernel::Kernel          src/04kernel/include/kernel/kernel.h:12-27
//   kernel::InfoCollector   src/04kernel/include/kernel/collector.h:10-24
#pragma once
#include <vector>
#include "runtime.h"

namespace refactor::hardware {
    struct Device {
        enum class Type { Cpu, Nvidia, Mlu };
    };
}// namespace refactor::hardware

namespace refactor::kernel {
    using runtime::Resources;
    using runtime::Routine;
    using RoutineWorkspace = runtime::Node;
    using Target = hardware::Device::Type;
    using Shape = std::vector<dim_t>;

    // host bytes of a constant tensor
    struct Blob {
        std::vector<uint8_t> bytes;
    };

    struct Tensor {
        DataType dataType;
        Shape shape;
        Arc<Blob> data;
        Tensor(DataType dt, Shape s, Arc<Blob> d = nullptr) noexcept : dataType(dt), shape(std::move(s)), data(std::move(d)) {}
        static Arc<Tensor> share(DataType dt, Shape s, Arc<Blob> d = nullptr) noexcept {
            return std::make_shared<Tensor>(dt, std::move(s), std::move(d));
        }
        int64_t rank() const { return static_cast<int64_t>(shape.size()); }
        size_t elementsSize() const {
            size_t n = 1;
            for (auto d : shape) n *= d;
            return n;
        }
        size_t bytesSize() const { return elementsSize() * dataType.size(); }
        void *malloc() {
            data = std::make_shared<Blob>();
            data->bytes.resize(bytesSize());
            return data->bytes.data();
        }
    };
    using TensorRefs = std::vector<std::reference_wrapper<Tensor const>>;

    class Kernel {
    public:
        virtual ~Kernel() = default;
        virtual size_t kernelTypeId() const = 0;
        virtual std::string_view description() const = 0;
        virtual RoutineWorkspace lower(Resources &) const { RUNTIME_ERROR("lower not implemented for this kernel"); }
        // Called once by the graph lowering, before lower(): isStatic[i] says that input i is a graph input which no node
        // of the graph writes (a weight).  A kernel may use it to fetch that operand while its predecessor still runs.
        virtual void hintStaticInputs(std::vector<bool> const &) {}
        template<class T, class... Args> bool is(Args &&...args) const noexcept {
            return this->kernelTypeId() == T::typeId(std::forward<Args>(args)...);
        }
    };
    using KernelBox = std::unique_ptr<Kernel>;

    class InfoCollector {
    protected:
        Target _target;
        constexpr explicit InfoCollector(Target target) : _target(target) {}

    public:
        virtual ~InfoCollector() = default;
        virtual std::vector<KernelBox> filter(TensorRefs inputs, TensorRefs outputs) const = 0;
    };
    using CollectorBox = std::unique_ptr<InfoCollector>;

}// namespace refactor::kernel
