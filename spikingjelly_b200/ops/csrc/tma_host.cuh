// Host-side helpers shared by the tensor-core kernels: the driver's tensor-map encoder, 2-D tensor maps for
// 16-bit and 8-bit row-major matrices, and the per-device status word that bounded waits report into.
#pragma once
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <cuda.h>
#include <cuda_runtime.h>

#include <vector>

namespace sjb200 {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = []() -> EncodeFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        TORCH_CHECK(e == cudaSuccess && q == cudaDriverEntryPointSuccess && p != nullptr,
                    "cuTensorMapEncodeTiled is not available from the driver");
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// 2-D map over a row-major [rows, cols] 16-bit matrix with `ld` elements per row; box = [box_rows, box_cols];
// box_cols * 2 bytes must equal the swizzle span (128 B or 64 B).
// Same for a [rows, cols] matrix of bytes (fp8): box = [box_rows, 128 bytes], 128-byte swizzle.
inline CUtensorMap make_map_u8(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "TMA: base address must be 16-byte aligned");
    TORCH_CHECK(ld % 16 == 0, "TMA: row pitch must be a multiple of 16 bytes (fp8 leading dimension % 16 == 0)");
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
    return m;
}

inline CUtensorMap make_map(const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, bool bf16, int box_cols = 64) {
    TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "TMA: base address must be 16-byte aligned");
    TORCH_CHECK((ld * 2) % 16 == 0, "TMA: row pitch must be a multiple of 16 bytes (leading dimension % 8 == 0)");
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    const CUtensorMapSwizzle sw = box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUresult r = encode_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
    return m;
}

inline at::Tensor& status_word(const at::Device& dev) {
    // deliberately leaked: tensors must not be destroyed after the CUDA context at process exit
    static auto* words = new std::vector<at::Tensor>(64);
    at::Tensor& w = (*words)[dev.index()];
    if (!w.defined()) w = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(dev));
    return w;
}


}  // namespace sjb200
