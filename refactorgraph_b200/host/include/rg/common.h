// Boundary types shared with the reference: DataType codes (src/00common/include/common/data_type.h:14-53),
// dim_t, and the error macros' behaviour (src/00common/include/common/error_handler.h:19-39:
// RUNTIME_ERROR/ASSERT -> std::runtime_error, TODO -> UnimplementError, UNREACHABLE -> UnreachableError).
#pragma once
#include <cstdint>
#include <memory>
#include <optional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace refactor {
    using dim_t = uint32_t;
    using ddim_t = int32_t;
    using count_t = uint32_t;
    template<class T> using Arc = std::shared_ptr<T>;

    struct UnimplementError : public std::logic_error {
        explicit UnimplementError(std::string m) : std::logic_error(std::move(m)) {}
    };
    struct UnreachableError : public std::logic_error {
        explicit UnreachableError(std::string m) : std::logic_error(std::move(m)) {}
    };
    inline std::string errorSite(char const *file, int line, std::string const &msg) {
        std::ostringstream s;
        s << msg << " Source " << file << ":" << line;
        return s.str();
    }
#define RUNTIME_ERROR(msg) throw std::runtime_error(::refactor::errorSite(__FILE__, __LINE__, (msg)))
#define ASSERT(cond, msg)                                                                        \
    do {                                                                                         \
        if (!(cond)) RUNTIME_ERROR(std::string("Assertion `" #cond "` failed with message: ") + (msg)); \
    } while (0)
#define UNREACHABLE() throw ::refactor::UnreachableError(::refactor::errorSite(__FILE__, __LINE__, "Unreachable."))
#define TODO(msg) throw ::refactor::UnimplementError(::refactor::errorSite(__FILE__, __LINE__, (msg)))

    struct DataType {
        enum : uint8_t {
            F32 = 1, U8 = 2, I8 = 3, U16 = 4, I16 = 5, I32 = 6, I64 = 7, String = 8, Bool = 9, FP16 = 10,
            F64 = 11, U32 = 12, U64 = 13, Complex64 = 14, Complex128 = 15, BF16 = 16,
        } internal;
        constexpr DataType(decltype(internal) i) noexcept : internal(i) {}
        constexpr operator decltype(internal)() const noexcept { return internal; }
        static std::optional<DataType> parse(uint8_t v) noexcept {
            if (v >= 1 && v <= 16) return DataType(static_cast<decltype(internal)>(v));
            return std::nullopt;
        }
        std::string_view name() const noexcept {
            static char const *N[] = {"", "F32", "U8", "I8", "U16", "I16", "I32", "I64", "String", "Bool", "FP16",
                                      "F64", "U32", "U64", "Complex64", "Complex128", "BF16"};
            return N[internal];
        }
        bool isFloat() const noexcept { return internal == F32 || internal == FP16 || internal == F64 || internal == BF16; }
        size_t size() const noexcept {
            switch (internal) {
                case U8: case I8: case Bool: return 1;
                case U16: case I16: case FP16: case BF16: return 2;
                case F32: case I32: case U32: return 4;
                case F64: case I64: case U64: case Complex64: return 8;
                case Complex128: return 16;
                default: return 0;
            }
        }
    };
}// namespace refactor
