// TEST INFRASTRUCTURE ONLY.  C entry points around the reference's own MX quantiser, so that the parity tests can
// run the reference's kernel itself (csrc/mxfp8_quantization.cu of the reference, compiled where it lies by
// oracle/Makefile into oracle/_ref/ with the reference's own nvcc flags) on the same inputs as this package's kernels.
// This file contains none of the reference's code: it declares the reference's two host functions
// (csrc/mxfp8_quantization.cu:229-246 and :267-284) and forwards to them.
#include <cuda_runtime.h>

namespace deepwell {
void quantize_to_mxfp8_bf16(void* output, void* scales, const void* input, int M, int N, bool row_major, cudaStream_t stream);
void dequantize_from_mxfp8_bf16(void* output, const void* input, const void* scales, int M, int N, bool row_major,
                                cudaStream_t stream);
}  // namespace deepwell

// output: int8 [M, N]; scales: fp32 [M, ceil(N / 32)]; input: bf16, row-major [M, N] or (row_major == 0) column-major.
extern "C" int ref_quantize_to_mxfp8_bf16(void* output, void* scales, const void* input, int M, int N, int row_major, void* stream) {
    deepwell::quantize_to_mxfp8_bf16(output, scales, input, M, N, row_major != 0, static_cast<cudaStream_t>(stream));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int ref_dequantize_from_mxfp8_bf16(void* output, const void* input, const void* scales, int M, int N, int row_major,
                                              void* stream) {
    deepwell::dequantize_from_mxfp8_bf16(output, input, scales, M, N, row_major != 0, static_cast<cudaStream_t>(stream));
    return static_cast<int>(cudaGetLastError());
}
