// Build-time stand-in used only when compiling the reference sources for the GPU baseline:
// the reference needs boost::filesystem::path (parent_path / filename / string) and boost is
// not installed, so the namespace is aliased to the C++17 standard library equivalent.
#pragma once
#include <filesystem>
namespace boost { namespace filesystem = std::filesystem; }
