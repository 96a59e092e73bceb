// Library-wide pieces of the C ABI: version, error text, device selection,
// the per-device status word and tensor-map encoding.
#include <cstring>
#include <mutex>

#include "host_util.h"
#include "ptx.cuh"

namespace tb {

// Written by kernels when a bounded wait runs out: [0] code, [1] CTA, [2] detail.
__device__ uint32_t g_status[4];

static thread_local char t_cuda_error[512] = "";

void set_cuda_error(const char* what, const char* file, int line) {
    snprintf(t_cuda_error, sizeof(t_cuda_error), "%s (%s:%d)", what, file, line);
}

static thread_local cudaEvent_t t_ev_before = nullptr, t_ev_after = nullptr;

void take_profile_events(cudaEvent_t* before, cudaEvent_t* after) {
    *before = t_ev_before;
    *after = t_ev_after;
    t_ev_before = t_ev_after = nullptr;
}

static std::mutex g_mu;
static constexpr int MAX_DEV = 64;
static int g_dev_state[MAX_DEV];  // 0 unknown, 1 ok, -1 unsupported
static int g_dev_sms[MAX_DEV];
static uint32_t* g_dev_status_ptr[MAX_DEV];

int select_device(int device, int* sm_count) {
    if (device < 0 || device >= MAX_DEV) return TB_ERR_BAD_ARG;
    TB_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev_state[device] == 0) {
        cudaDeviceProp prop;
        TB_CUDA(cudaGetDeviceProperties(&prop, device));
        g_dev_sms[device] = prop.multiProcessorCount;
        if (prop.major != 10) {
            g_dev_state[device] = -1;
        } else {
            void* p = nullptr;
            TB_CUDA(cudaGetSymbolAddress(&p, g_status));
            g_dev_status_ptr[device] = static_cast<uint32_t*>(p);
            TB_CUDA(cudaMemset(p, 0, sizeof(uint32_t) * 4));
            g_dev_state[device] = 1;
        }
    }
    if (g_dev_state[device] < 0) return TB_ERR_UNSUPPORTED;
    if (sm_count) *sm_count = g_dev_sms[device];
    return TB_OK;
}

uint32_t* status_ptr(int device) { return g_dev_status_ptr[device]; }

// One CTA waits, with the kernels' own bounded wait, on an mbarrier that nothing will ever arrive
// at; when the limit runs out it records the failure exactly as the pipelines do and returns.
__global__ void selftest_wait_kernel(uint32_t* status, uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_word = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        volatile uint32_t* abort_flag = &abort_word;
        if (!mbar_wait(smem_u32(&bar), 0u, abort_flag, limit_ns)) {
            if (atomicCAS(status, 0u, (uint32_t)ST_TIMEOUT_EMPTY) == 0u) {
                status[1] = 0xFFFFFFFFu;  // marks the self-test
                status[2] = 0;
            }
        }
    }
    __syncthreads();
}

typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);
static encode_fn g_encode = nullptr;

int encode_tmap(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swizzle) {
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            TB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
            if (!fn || qres != cudaDriverEntryPointSuccess) {
                set_cuda_error("cuTensorMapEncodeTiled not available", __FILE__, __LINE__);
                return TB_ERR_CUDA;
            }
            g_encode = reinterpret_cast<encode_fn>(fn);
        }
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bdim[5], estr[5];
    for (uint32_t i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUresult r = g_encode(map, dt, rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[96];
        snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        set_cuda_error(msg, __FILE__, __LINE__);
        return TB_ERR_CUDA;
    }
    return TB_OK;
}

}  // namespace tb

extern "C" {

int tb_version(void) { return 100; }

const char* tb_strerror(int code) {
    switch (code) {
    case TB_OK: return "ok";
    case TB_ERR_BAD_DTYPE: return "unsupported dtype (expected fp16, bf16 or fp32)";
    case TB_ERR_BAD_SHAPE: return "invalid shape or leading dimension";
    case TB_ERR_BAD_PROJ_DIM: return "Invalid Number of JL dimensions it has to be a multiple of 512";
    case TB_ERR_BAD_ARG: return "invalid argument";
    case TB_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case TB_ERR_CUDA: return "CUDA error";
    case TB_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case TB_ERR_UNSUPPORTED: return "unsupported device or size";
    case TB_ERR_NOT_SPD: return "matrix is not positive definite (non-positive Cholesky pivot)";
    case TB_ERR_SCRATCH_LIMIT:
        return "shape needs more scratch than tb_project_static's built-in array; use tb_project with a workspace";
    default: return "unknown error code";
    }
}

const char* tb_last_cuda_error(void) { return tb::t_cuda_error; }

int tb_profile_events(void* before, void* after) {
    tb::t_ev_before = static_cast<cudaEvent_t>(before);
    tb::t_ev_after = static_cast<cudaEvent_t>(after);
    return TB_OK;
}

int tb_selftest_wait_timeout(int device, void* stream, uint32_t limit_ms) {
    if (limit_ms == 0 || limit_ms > 2000) return TB_ERR_BAD_ARG;
    int rc = tb::select_device(device, nullptr);
    if (rc != TB_OK) return rc;
    tb::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(tb::status_ptr(device),
                                                                              (uint64_t)limit_ms * 1000000ull);
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_device_status(int device, uint32_t* detail) {
    int rc = tb::select_device(device, nullptr);
    if (rc != TB_OK) return rc;
    uint32_t host[4] = {0, 0, 0, 0};
    TB_CUDA(cudaDeviceSynchronize());
    TB_CUDA(cudaMemcpy(host, tb::status_ptr(device), sizeof(host), cudaMemcpyDeviceToHost));
    if (detail) *detail = host[0];
    if (host[0] != 0) {
        TB_CUDA(cudaMemset(tb::status_ptr(device), 0, sizeof(host)));
        return host[0] == 6u ? TB_ERR_NOT_SPD : TB_ERR_DEVICE_TIMEOUT;
    }
    return TB_OK;
}

}  // extern "C"
