// Test-infrastructure shim, found ahead of the reference's 3rdparty/utils/cuda_utils.h when the
// reference quantizer (3rdparty/cutlass_kernels/cutlass_preprocessors.cc) is compiled for the host
// as a checking oracle.  It supplies the two assertion macros that file uses and a getSMVersion()
// that does not touch the CUDA runtime: the real one (3rdparty/utils/cuda_utils.h:63-72) calls
// cudaGetDevice, which fails on a machine without a GPU and reports 100 on a B200, where the
// reference packer rejects the architecture (cutlass_preprocessors.cc:113-127).  80 selects the
// sm75-89 packing the reference was written for.
#pragma once
#include <stdexcept>
#include <string>

#include "string_utils.h"  // the reference's fmtstr(), reached through its own include path

namespace fastertransformer {

inline void oracle_shim_assert(bool ok, const char* file, int line, const std::string& info = "")
{
    if (!ok) {
        throw std::runtime_error(std::string("[oracle/_ref] ") + info + " assertion failed: " + file + ":"
                                 + std::to_string(line));
    }
}

#define FT_CHECK(val) fastertransformer::oracle_shim_assert((val), __FILE__, __LINE__)
#define FT_CHECK_WITH_INFO(val, info) fastertransformer::oracle_shim_assert((val), __FILE__, __LINE__, (info))

inline int getSMVersion()
{
    return 80;
}

}  // namespace fastertransformer
