// Epilogue of finalize_scores on the device (trak/traker.py:676-678):
//
//     out[r, c] = (score_sum[r, c] / M) * (out_to_loss_sum[r] / M)
//
// score_sum is the sum over M checkpoints of the per-checkpoint score products, out_to_loss_sum
// the sum of the per-checkpoint out-to-loss weights.  The reference does this with numpy on the
// host over the whole [n_train, n_targets] array; here it is one HBM-bound pass over a row block
// that is still on the GPU, writing fp32 or fp16 (the dtype of the scores store), so the block
// leaves the device once, finished.  Both divisions are true IEEE divisions and the product is a
// single rounded multiply, i.e. the same three fp32 operations numpy performs.
#include <cuda_fp16.h>

#include "host_util.h"

namespace tb {

template <typename Out>
__global__ void finalize_scores_kernel(const float* __restrict__ acc, int64_t ld_acc,
                                       const float* __restrict__ w_sum, int64_t n, int64_t m, float num_models,
                                       Out* __restrict__ out, int64_t ld_out) {
    // a thread handles 4 consecutive targets of one train row: one 16-byte load and, where the output row is
    // aligned for it, one 16-byte (fp32) or 8-byte (fp16) store; m4 = ceil(m / 4)
    const int64_t m4 = (m + 3) / 4;
    const int64_t total = n * m4;
    const bool vec_in = (ld_acc % 4) == 0 && (reinterpret_cast<uintptr_t>(acc) & 15u) == 0;
    const bool vec_out = (ld_out % 4) == 0 && (reinterpret_cast<uintptr_t>(out) & (4u * sizeof(Out) - 1u)) == 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / m4, c = (i % m4) * 4;
        const float w = __fdiv_rn(w_sum[r], num_models);
        const float* src = acc + r * ld_acc + c;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const bool whole = c + 4 <= m;
        if (vec_in && whole) {
            const float4 x = *reinterpret_cast<const float4*>(src);
            v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        } else {
            for (int e = 0; e < 4 && c + e < m; ++e) v[e] = src[e];
        }
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = __fmul_rn(__fdiv_rn(v[e], num_models), w);
        Out* dst = out + r * ld_out + c;
        if (vec_out && whole) {
            if constexpr (sizeof(Out) == 2) {
                const __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
                uint2 o;
                o.x = *reinterpret_cast<const uint32_t*>(&lo);
                o.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = o;
            } else {
                *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
            }
        } else {
            for (int e = 0; e < 4 && c + e < m; ++e) {
                if constexpr (sizeof(Out) == 2)
                    dst[e] = __float2half_rn(y[e]);
                else
                    dst[e] = y[e];
            }
        }
    }
}

}  // namespace tb

extern "C" int tb_finalize_scores(int device, void* stream_, const float* score_sum, int64_t ld_sum,
                                  const float* out_to_loss_sum, int64_t n, int64_t m, float num_models, void* out,
                                  int out_dtype, int64_t ld_out) {
    using namespace tb;
    if (out_dtype != TB_F16 && out_dtype != TB_F32) return TB_ERR_BAD_DTYPE;
    if (n <= 0 || m <= 0 || ld_sum < m || ld_out < m) return TB_ERR_BAD_SHAPE;
    if (!score_sum || !out_to_loss_sum || !out || !(num_models > 0.0f)) return TB_ERR_BAD_ARG;
    int sm_count = 0;
    int rc = select_device(device, &sm_count);
    if (rc != TB_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t total = n * ((m + 3) / 4);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 32;
    if (blocks > cap) blocks = cap;
    if (out_dtype == TB_F16)
        finalize_scores_kernel<__half><<<(uint32_t)blocks, 256, 0, stream>>>(
            score_sum, ld_sum, out_to_loss_sum, n, m, num_models, static_cast<__half*>(out), ld_out);
    else
        finalize_scores_kernel<float><<<(uint32_t)blocks, 256, 0, stream>>>(
            score_sum, ld_sum, out_to_loss_sum, n, m, num_models, static_cast<float*>(out), ld_out);
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}
