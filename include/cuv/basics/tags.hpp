// Memory-space and layout tags (basics/tags.hpp:13-20, basics/memory.hpp:32-36 in CUV).
#pragma once
namespace cuv {
struct host_memory_space {};
struct dev_memory_space {};
struct row_major {};
struct column_major {};
}  // namespace cuv
