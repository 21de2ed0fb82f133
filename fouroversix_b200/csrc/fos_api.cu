// Library-wide entry points: version, status strings, device check.
#include "fos_common.cuh"

namespace fos {

static thread_local int g_last_cuda_error = 0;

int note_cuda_error(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    return FOS_ERR_CUDA;
}

int check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return note_cuda_error(e);
    // one attribute query per call is cheap (no context switch), and stays correct when the
    // caller moves between devices
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return note_cuda_error(e);
    return major == 10 ? FOS_OK : FOS_ERR_ARCH;
}

}  // namespace fos

extern "C" int fos_version(void) { return 200; }

extern "C" int fos_wait_failure_site(int32_t *site) {
    if (!site) return FOS_ERR_INVALID_ARGUMENT;
    int32_t q = 0, g = 0, f = 0;
    FOS_CUDA_TRY(fos::quantize_wait_failures(&q));
    FOS_CUDA_TRY(fos::gemm_wait_failures(&g));
    FOS_CUDA_TRY(fos::gemm_if4_wait_failures(&f));
    *site = q != 0 ? q : (g != 0 ? 100 + g : (f != 0 ? 200 + f : 0));
    return FOS_OK;
}

extern "C" int fos_wait_failure_roles(uint32_t roles[3]) {
    if (!roles) return FOS_ERR_INVALID_ARGUMENT;
    FOS_CUDA_TRY(fos::quantize_wait_roles(&roles[0]));
    FOS_CUDA_TRY(fos::gemm_wait_roles(&roles[1]));
    FOS_CUDA_TRY(fos::gemm_if4_wait_roles(&roles[2]));
    return FOS_OK;
}

extern "C" int fos_last_cuda_error(void) { return fos::g_last_cuda_error; }

extern "C" const char *fos_status_string(int status) {
    switch (status) {
        case FOS_OK: return "ok";
        case FOS_ERR_INVALID_ARGUMENT: return "invalid argument";
        case FOS_ERR_UNSUPPORTED: return "unsupported combination of options";
        case FOS_ERR_MISALIGNED: return "pointer or stride is not aligned as required";
        case FOS_ERR_CUDA: return "a CUDA runtime call failed";
        case FOS_ERR_ARCH: return "the current device is not compute capability 10.x (B200)";
        case FOS_ERR_TIMEOUT: return "a bounded device-side wait timed out";
        case FOS_ERR_TOO_LARGE: return "size beyond the documented maximum";
        default: return "unknown status";
    }
}
