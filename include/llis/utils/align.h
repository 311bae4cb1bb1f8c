#pragma once
#include <cstddef>
namespace llis {
namespace utils {
// Smallest multiple of `align` that is >= pos (reference: include/llis/utils/align.h:11-13).
constexpr size_t next_aligned_pos(size_t pos, size_t align) { return (pos + align - 1) / align * align; }
}  // namespace utils
}  // namespace llis
