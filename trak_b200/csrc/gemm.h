// Internal interface of the tensor-core GEMM (gemm.cu) for the other translation units.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace tb {

// A packed operand: [128-row block][32-wide k block][plane][128 rows][32 k], 16-bit elements
// (data_bytes).  fp32 sources (`scaled`) become two planes, fp16 hi / lo of the value times a
// per-row power of two; their tiles are followed by one 32-bit word per packed row, the bit
// pattern of the row's largest magnitude, which fixes that scale.
struct Packed {
    uint32_t rowblocks, kblocks, npl;
    bool scaled;
    size_t data_bytes, bytes;
};
inline uint32_t* packed_amax(const uint16_t* packed, const Packed& g) {
    return reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(const_cast<uint16_t*>(packed)) + g.data_bytes);
}

Packed packed_geometry(int dtype, int64_t rows, int64_t K);

// Packs `rows` x `K` operand elements from a row-major source (transposed when `trans`).
int launch_pack(const void* src, int dtype, bool trans, uint64_t rows, uint64_t K, uint64_t ld,
                uint16_t* packed, const Packed& g, int sm_count, cudaStream_t stream);

// C[M x N] (+)= alpha * row_scale[m] * Apacked . Bpacked^T  (symmetric: A == B, mirrored stores;
// chunked: scaled fp32 operands only -- the tensor core accumulates 64 k at a time and the chunks are
// summed with rounded fp32 adds, for products whose error an inverse will amplify)
int launch_gemm(int device, cudaStream_t stream, const uint16_t* pa, const Packed& ga, const uint16_t* pb,
                const Packed& gb, int dtype, int64_t M, int64_t N, float* C, int64_t ldc,
                const float* row_scale, float alpha, int accumulate, int symmetric, int chunked);

}  // namespace tb
