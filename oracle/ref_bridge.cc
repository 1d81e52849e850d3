// Test infrastructure: C entry points around the UNMODIFIED reference quantizer and packer, which the
// Makefile beside this file compiles from the reference checkout where it lies.  Only tests, the
// smoke check and the CPU-baseline leg of the benchmark load the resulting library; the product never
// does.
//
// Wrapped reference functions (3rdparty/cutlass_kernels/cutlass_preprocessors.cc):
//   symmetric_quantize<half,half>   / <float,float>  (:581-678), the 6-argument overload that also
//   returns the row-major, un-packed int8 matrix;  preprocess_weights (:536-544).
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>
#include <exception>
#include <vector>

#include "cutlass_kernels/cutlass_preprocessors.h"

namespace ft = fastertransformer;

extern "C" {

// weight: row-major [rows=K, cols=N]; dtype_is_fp32 selects the <float,float> instantiation (scales
// fp32) else <half,half> (scales fp16) exactly as fpA_intB_gemm_wrapper.cu:76-93 does.
int ref_symmetric_quantize_int8(const void* weight, int dtype_is_fp32, size_t rows, size_t cols,
                                int8_t* unprocessed, int8_t* processed, void* scales)
{
    try {
        std::vector<size_t> shape{rows, cols};
        if (dtype_is_fp32) {
            ft::symmetric_quantize<float, float>(processed, unprocessed, reinterpret_cast<float*>(scales),
                                                 reinterpret_cast<const float*>(weight), shape,
                                                 ft::QuantType::INT8_WEIGHT_ONLY);
        }
        else {
            ft::symmetric_quantize<half, half>(processed, unprocessed, reinterpret_cast<half*>(scales),
                                               reinterpret_cast<const half*>(weight), shape,
                                               ft::QuantType::INT8_WEIGHT_ONLY);
        }
    }
    catch (const std::exception& e) {
        std::fprintf(stderr, "ref_symmetric_quantize_int8: %s\n", e.what());
        return 1;
    }
    return 0;
}

int ref_preprocess_weights_int8(const int8_t* row_major, size_t rows, size_t cols, int arch, int8_t* processed)
{
    try {
        ft::preprocess_weights(processed, row_major, rows, cols, /*is_int4=*/false, arch);
    }
    catch (const std::exception& e) {
        std::fprintf(stderr, "ref_preprocess_weights_int8: %s\n", e.what());
        return 1;
    }
    return 0;
}

}  // extern "C"
