// Build shim for the reference oracle: the reference uses absl::InlinedVector only as a
// small-size-optimised std::vector. abseil is not vendored, so a std::vector subclass stands in.
#pragma once
#include <cstddef>
#include <memory>
#include <vector>
namespace absl {
    template<class T, std::size_t N, class A = std::allocator<T>>
    class InlinedVector : public std::vector<T, A> {
    public:
        using std::vector<T, A>::vector;
    };
}// namespace absl
