// tb_project_static: the JL projection for callers that cannot hand the library a
// workspace of their own.
//
// tb_project needs scratch memory (the restaged 16-bit copy of the gradients and the
// per-bundle fp32 partials) and leaves its allocation to the caller.  Some callers have
// nowhere to get it from: a C host embedded in a process whose device memory has been
// handed out in full to another component's pool, or a latency-critical loop that must
// not run into the device-wide synchronisation a cudaMalloc / cudaFree implies.  For them
// this entry point keeps the scratch in a fixed array that is part of the loaded module.
// Nothing is allocated here or anywhere below it: no cudaMalloc, no cudaFree, no library
// routine that allocates.
#include <mutex>

#include "host_util.h"

namespace tb {

// The scratch itself.  Every GPU that loads the library holds these bytes until the
// process exits, so the size is deliberately modest.
constexpr size_t STATIC_SCRATCH_BYTES = TB_PROJECT_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_project_scratch[STATIC_SCRATCH_BYTES];

static std::mutex g_scratch_mu;
static void* g_scratch_ptr[64];  // device address of g_project_scratch, per device

// In host code the array's name is only a handle for the runtime, not a device address.
// The address is looked up once per device, with that device current (select_device has made it
// so).  With the runtime's lazy module loading this look-up can be the moment the driver sets
// the array's bytes aside on that GPU, so it can fail for lack of memory; a failure is reported,
// not remembered, and leaves no error pending in the runtime.
static int scratch_address(int device, void** out) {
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_ptr[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_project_scratch);
        if (e != cudaSuccess || !p) {
            set_cuda_error(e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned a null address",
                           __FILE__, __LINE__);
            (void)cudaGetLastError();  // do not let a later launch check report this failure
            return TB_ERR_CUDA;
        }
        g_scratch_ptr[device] = p;
    }
    *out = g_scratch_ptr[device];
    return TB_OK;
}

}  // namespace tb

extern "C" int tb_project_static(int device, void* stream, const void* grads, int dtype, int64_t B,
                                 int64_t F, int64_t ld, float* out, int64_t ld_out, uint32_t N,
                                 uint32_t seed, uint32_t num_feature_tiles, int proj_type, float alpha,
                                 int accumulate) {
    // Same argument rules and codes as tb_project, checked before the device is touched.
    int rc = tb::validate_project_args(grads, dtype, B, F, ld, out, ld_out, N, num_feature_tiles, proj_type);
    if (rc != TB_OK) return rc;
    // Shapes whose scratch does not fit the fixed array are refused up front.
    const size_t need = tb_project_workspace_bytes(dtype, B, F, N, num_feature_tiles);
    if (need > tb::STATIC_SCRATCH_BYTES) return TB_ERR_SCRATCH_LIMIT;
    // Makes `device` current and refuses anything that is not a B200-class GPU.
    rc = tb::select_device(device, nullptr);
    if (rc != TB_OK) return rc;
    void* scratch = nullptr;
    rc = tb::scratch_address(device, &scratch);
    if (rc != TB_OK) return rc;
    // Every scratch byte the kernels read (staged gradients including their zero padding,
    // partial sums) is written earlier in the same call, so nothing has to start at zero
    // and the previous call's leftovers are harmless.
    return tb_project(device, stream, grads, dtype, B, F, ld, out, ld_out, N, seed, num_feature_tiles,
                      proj_type, alpha, accumulate, scratch, tb::STATIC_SCRATCH_BYTES);
}
